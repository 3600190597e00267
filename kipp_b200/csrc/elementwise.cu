// Embedding gather, RMSNorm, layer norm, PolyNorm and element-wise activations.
//
// Reference counterparts: embed_kernel (cuda/kipp_kernels.cu:35) handles one
// token per launch, rms_norm_kernel (cuda/kipp_kernels.cu:44) one row in one
// block.  These take any number of tokens / rows per launch.
#include "common.cuh"
#include <algorithm>

// out[t, :] = float(table[ids[t], :]).  The residual stream is float32.
template <typename TW>
__global__ void embed_gather_kernel(float* __restrict__ out, const TW* __restrict__ table,
                                    const int* __restrict__ ids, int hidden, int vocab,
                                    int* __restrict__ status) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    if (id < 0 || id >= vocab) {           // never read outside the table
        if (threadIdx.x == 0) atomicExch(status, 1);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)t * hidden + i] = 0.f;
        return;
    }
    const TW* row = table + (size_t)id * hidden;
    float* dst = out + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32(row[i]);
}

extern "C" int kipp_embed_gather(float* out, const void* table, int table_dtype, const int* ids,
                                 int tokens, int hidden, int vocab, int* status, void* stream) {
    if (tokens <= 0) return 0;
    if (hidden <= 0 || vocab <= 0) return KIPP_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == KIPP_DT_F32)
        return kipp_launch(embed_gather_kernel<float>, dim3(tokens), dim3(threads), 0, s, 1, out,
                           (const float*)table, ids, hidden, vocab, status);
    if (table_dtype == KIPP_DT_BF16)
        return kipp_launch(embed_gather_kernel<bf16>, dim3(tokens), dim3(threads), 0, s, 1, out,
                           (const bf16*)table, ids, hidden, vocab, status);
    return KIPP_ERR_DTYPE;
}

// y[r, i] = x[src(r), i] * rsqrt(mean(x[src(r), :]^2) + eps) * w[i]
// (src/kipp.c:2221-2231).  Sum of squares and scale in float32.  `rows`, when
// not null, gathers the input rows (used for the rows whose logits are wanted).
template <typename TO>
__global__ void rmsnorm_kernel(TO* __restrict__ out, const float* __restrict__ x,
                               const void* __restrict__ w, int w_dtype, const int* __restrict__ rows,
                               int size, float eps, float* __restrict__ ssq_out) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* src = x + (size_t)(rows ? rows[r] : r) * size;
    float ss = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float v = src[i];
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    // deferred form: x * w alone goes out, the sum of squares beside it (see kipp_rmsnorm_deferred)
    const float scale = ssq_out ? 1.0f : 1.0f / sqrtf(ss / (float)size + eps);
    if (ssq_out && threadIdx.x == 0) ssq_out[r] = ss;
    TO* dst = out + (size_t)r * size;
    for (int i = threadIdx.x; i < size; i += blockDim.x)
        dst[i] = from_f32<TO>(src[i] * scale * load_w(w, w_dtype, i));
}

// Vector path: size a multiple of 4 and at most 4096; each of 256 threads keeps
// its float4 pieces of the row in registers, so the row is read once.
template <typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_vec_kernel(TO* __restrict__ out, const float* __restrict__ x, const void* __restrict__ w, int w_dtype,
                   const int* __restrict__ rows, int size, float eps, float* __restrict__ ssq_out) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * size);
    const int n4 = size >> 2;
    float4 v[4];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = threadIdx.x + 256 * j;
        if (i < n4) {
            v[j] = src[i];
            ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        }
    }
    ss = block_sum(ss, scratch);
    const float scale = ssq_out ? 1.0f : 1.0f / sqrtf(ss / (float)size + eps);
    if (ssq_out && threadIdx.x == 0) ssq_out[r] = ss;
    TO* dst = out + (size_t)r * size;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = threadIdx.x + 256 * j;
        if (i < n4) {
            const size_t e = (size_t)i * 4;
            const float a = v[j].x * scale * load_w(w, w_dtype, e), b = v[j].y * scale * load_w(w, w_dtype, e + 1);
            const float c = v[j].z * scale * load_w(w, w_dtype, e + 2), d = v[j].w * scale * load_w(w, w_dtype, e + 3);
            if (sizeof(TO) == 4) {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + e) = make_float4(a, b, c, d);
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
                uint2 packed;
                packed.x = *reinterpret_cast<uint32_t*>(&lo);
                packed.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(dst) + e) = packed;
            }
        }
    }
}

static int rmsnorm_launch(void* out, int out_dtype, const float* x, const void* w, int w_dtype, const int* rows,
                          int n_rows, int size, float eps, float* ssq_out, void* stream) {
    if (n_rows <= 0) return 0;
    if (size <= 0) return KIPP_ERR_ARG;
    if (w_dtype != KIPP_DT_F32 && w_dtype != KIPP_DT_BF16) return KIPP_ERR_DTYPE;
    cudaStream_t s = (cudaStream_t)stream;
    if (size % 4 == 0 && size <= 4096 && size >= 256 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        if (out_dtype == KIPP_DT_F32)
            return kipp_launch(rmsnorm_vec_kernel<float>, dim3(n_rows), dim3(256), 0, s, 1, (float*)out, x, w,
                               w_dtype, rows, size, eps, ssq_out);
        if (out_dtype == KIPP_DT_BF16)
            return kipp_launch(rmsnorm_vec_kernel<bf16>, dim3(n_rows), dim3(256), 0, s, 1, (bf16*)out, x, w,
                               w_dtype, rows, size, eps, ssq_out);
        return KIPP_ERR_DTYPE;
    }
    int threads = size >= 2048 ? 512 : (size >= 512 ? 256 : 64);
    if (out_dtype == KIPP_DT_F32)
        return kipp_launch(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, s, 1, (float*)out, x, w, w_dtype,
                           rows, size, eps, ssq_out);
    if (out_dtype == KIPP_DT_BF16)
        return kipp_launch(rmsnorm_kernel<bf16>, dim3(n_rows), dim3(threads), 0, s, 1, (bf16*)out, x, w, w_dtype,
                           rows, size, eps, ssq_out);
    return KIPP_ERR_DTYPE;
}

extern "C" int kipp_rmsnorm(void* out, int out_dtype, const float* x, const void* w, int w_dtype,
                            const int* rows, int n_rows, int size, float eps, void* stream) {
    return rmsnorm_launch(out, out_dtype, x, w, w_dtype, rows, n_rows, size, eps, nullptr, stream);
}

// The norm with its per-row factor left to whoever reads the result: out[r, i] = x[row r, i] * w[i]
// (rounded to out's type) and ssq_out[r] = sum of x[row r, :]^2, so that
// rmsnorm(x)[r] = out[r] / sqrt(ssq_out[r] / size + eps).  A matrix product that follows applies
// the factor to its own result rows in float32 (kipp_gemm_tc_fold); a residual add that leaves
// x * w itself (the same kernel library) rounds the same values the same way, so both routes to
// the product's input agree to the bit.
extern "C" int kipp_rmsnorm_deferred(void* out, int out_dtype, float* ssq_out, const float* x, const void* w,
                                     int w_dtype, const int* rows, int n_rows, int size, void* stream) {
    if (ssq_out == nullptr) return KIPP_ERR_ARG;
    return rmsnorm_launch(out, out_dtype, x, w, w_dtype, rows, n_rows, size, 0.f, ssq_out, stream);
}

// ---------------------------------------------------------------------------
// PolyNorm activation over each row of z [rows, n]:
//   y = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3,
// powers taken element by element, N(x) = x / sqrt(mean(x^2) + eps) over the
// row.  The three mean squares (of z, z^2 and z^3) and the polynomial are
// float32; z arrives and y leaves in the compute type.  One block per row.
template <typename T>
__global__ void __launch_bounds__(256)
polynorm_kernel(T* __restrict__ out, long long ld_out, const T* __restrict__ z, long long ld_z,
                const float* __restrict__ coef, int n, float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const T* src = z + (size_t)blockIdx.x * ld_z;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = to_f32(src[i]);
        const float v2 = v * v, v3 = v2 * v;
        s2 += v2;
        s4 = fmaf(v2, v2, s4);
        s6 = fmaf(v3, v3, s6);
    }
    s2 = block_sum(s2, scratch);
    s4 = block_sum(s4, scratch);
    s6 = block_sum(s6, scratch);
    const float inv_n = 1.0f / (float)n;
    const float r1 = coef[0] / sqrtf(s2 * inv_n + eps), r2 = coef[1] / sqrtf(s4 * inv_n + eps);
    const float r3 = coef[2] / sqrtf(s6 * inv_n + eps), c3 = coef[3];
    T* dst = out + (size_t)blockIdx.x * ld_out;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = to_f32(src[i]);
        const float v2 = v * v;
        dst[i] = from_f32<T>(fmaf(r1, v, fmaf(r2, v2, fmaf(r3, v2 * v, c3))));
    }
}

extern "C" int kipp_polynorm(void* out, long long ld_out, const void* z, long long ld_z, int dtype,
                             const float* coef, int rows, int n, float eps, void* stream) {
    if (rows <= 0) return 0;
    if (n <= 0 || coef == nullptr) return KIPP_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = n >= 1024 ? 256 : 128;
    if (dtype == KIPP_DT_F32)
        return kipp_launch(polynorm_kernel<float>, dim3(rows), dim3(threads), 0, s, 1, (float*)out, ld_out,
                           (const float*)z, ld_z, coef, n, eps);
    if (dtype == KIPP_DT_BF16)
        return kipp_launch(polynorm_kernel<bf16>, dim3(rows), dim3(threads), 0, s, 1, (bf16*)out, ld_out,
                           (const bf16*)z, ld_z, coef, n, eps);
    return KIPP_ERR_DTYPE;
}

// x += y over n float32 values (the embedding output fed back into the residual stream).
__global__ void add_f32_kernel(float* __restrict__ x, const float* __restrict__ y, long long n) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += y[i];
}

extern "C" int kipp_add_f32(float* x, const float* y, long long n, void* stream) {
    if (n <= 0) return 0;
    const long long blocks = (n + 255) / 256;
    if (blocks > 0x7fffffffLL) return KIPP_ERR_ARG;
    return kipp_launch(add_f32_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, 1, x, y, n);
}

// ---------------------------------------------------------------------------
// Layer norm with weight and bias: y[r, i] = (x[src(r), i] - mean) / sqrt(var + eps) * w[i] + b[i],
// var = the mean of the squared deviations (two passes over the row, which a block keeps in
// shared memory), all of it float32.  `rows`, when not null, gathers the input rows; b may be null.
template <typename TO>
__global__ void __launch_bounds__(256)
layernorm_kernel(TO* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                 const float* __restrict__ b, const int* __restrict__ rows, int size, float eps) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* src = x + (size_t)(rows ? rows[r] : r) * size;
    float s = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float v = src[i];
        row[i] = v;
        s += v;
    }
    const float mean = block_sum(s, scratch) / (float)size;
    float ss = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float d = row[i] - mean;
        ss = fmaf(d, d, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)size + eps);
    TO* dst = out + (size_t)r * size;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float y = (row[i] - mean) * inv * w[i];
        dst[i] = from_f32<TO>(b ? y + b[i] : y);
    }
}

extern "C" int kipp_layernorm(void* out, int out_dtype, const float* x, const float* w, const float* b,
                              const int* rows, int n_rows, int size, float eps, void* stream) {
    if (n_rows <= 0) return 0;
    if (size <= 0 || size > 48 * 1024 / 4 || w == nullptr) return KIPP_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = size >= 1024 ? 256 : 128;
    const size_t smem = (size_t)size * sizeof(float);
    if (out_dtype == KIPP_DT_F32)
        return kipp_launch(layernorm_kernel<float>, dim3(n_rows), dim3(threads), smem, s, 1, (float*)out, x, w, b, rows,
                           size, eps);
    if (out_dtype == KIPP_DT_BF16)
        return kipp_launch(layernorm_kernel<bf16>, dim3(n_rows), dim3(threads), smem, s, 1, (bf16*)out, x, w, b, rows,
                           size, eps);
    return KIPP_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// Activations applied element by element to z [rows, n] in the compute type, arithmetic in
// float32: 0 relu, 1 the square of relu, 2 gelu with the tanh form
// 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), 3 silu.
template <typename T>
__global__ void activation_kernel(T* __restrict__ out, long long ld_out, const T* __restrict__ z, long long ld_z,
                                  int rows, int n, int kind) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * n) return;
    const long long r = i / n, c = i % n;
    out[r * ld_out + c] = from_f32<T>(kipp_activation(to_f32(z[r * ld_z + c]), kind));
}

extern "C" int kipp_activation(void* out, long long ld_out, const void* z, long long ld_z, int dtype, int rows,
                               int n, int kind, void* stream) {
    if (rows <= 0 || n <= 0) return 0;
    if (kind < 0 || kind > 3) return KIPP_ERR_ARG;
    const long long total = (long long)rows * n, blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) return KIPP_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == KIPP_DT_F32)
        return kipp_launch(activation_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, s, 1, (float*)out, ld_out,
                           (const float*)z, ld_z, rows, n, kind);
    if (dtype == KIPP_DT_BF16)
        return kipp_launch(activation_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, s, 1, (bf16*)out, ld_out,
                           (const bf16*)z, ld_z, rows, n, kind);
    return KIPP_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// A second embedding table addressed by a hash of the token pair: x[t, :] += table[row(t), :] with
// row = (previous token * mul_prev + token * mul_cur) mod buckets, and row = buckets (the table's
// extra last row) for the token at position 0 of its sequence.  The previous token of a step's
// first token is the one the sequence's slot keeps (last_token[slot * stride], written by
// kipp_keep_last_token after this kernel: the token before is part of a sequence's state).
template <typename TW>
__global__ void hashed_pair_add_kernel(float* __restrict__ x, const TW* __restrict__ table,
                                       const int* __restrict__ ids, const int* __restrict__ positions,
                                       const int* __restrict__ entry_of_token, const int* __restrict__ q_start,
                                       const int* __restrict__ slots, const int* __restrict__ last_token,
                                       long long stride, int hidden, int vocab, long long buckets, long long mul_prev,
                                       long long mul_cur, int* __restrict__ status) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t], e = entry_of_token[t];
    long long row = buckets;
    if (positions[t] > 0) {
        const int prev = t > q_start[e] ? ids[t - 1] : last_token[(size_t)slots[e] * stride];
        if (id < 0 || id >= vocab || prev < 0 || prev >= vocab) {      // never read outside the table
            if (threadIdx.x == 0) atomicExch(status, 1);
            return;
        }
        row = ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
    }
    const TW* src = table + (size_t)row * hidden;
    float* dst = x + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] += to_f32(src[i]);
}

extern "C" int kipp_hashed_pair_add(float* x, const void* table, int table_dtype, const int* ids, const int* positions,
                                    const int* entry_of_token, const int* q_start, const int* slots,
                                    const int* last_token, long long stride, int tokens, int hidden, int vocab,
                                    long long buckets, long long mul_prev, long long mul_cur, int* status, void* stream) {
    if (tokens <= 0) return 0;
    if (hidden <= 0 || vocab <= 0 || buckets <= 0 || mul_prev < 0 || mul_cur < 0 || last_token == nullptr || stride <= 0)
        return KIPP_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == KIPP_DT_F32)
        return kipp_launch(hashed_pair_add_kernel<float>, dim3(tokens), dim3(threads), 0, s, 1, x, (const float*)table, ids,
                           positions, entry_of_token, q_start, slots, last_token, stride, hidden, vocab, buckets, mul_prev,
                           mul_cur, status);
    if (table_dtype == KIPP_DT_BF16)
        return kipp_launch(hashed_pair_add_kernel<bf16>, dim3(tokens), dim3(threads), 0, s, 1, x, (const bf16*)table, ids,
                           positions, entry_of_token, q_start, slots, last_token, stride, hidden, vocab, buckets, mul_prev,
                           mul_cur, status);
    return KIPP_ERR_DTYPE;
}

// last_token[slots[e] * stride] = the last token entry e brings in this step.
__global__ void keep_last_token_kernel(int* __restrict__ last_token, long long stride, const int* __restrict__ ids,
                                       const int* __restrict__ q_start, const int* __restrict__ slots, int entries) {
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e < entries && q_start[e + 1] > q_start[e]) last_token[(size_t)slots[e] * stride] = ids[q_start[e + 1] - 1];
}

extern "C" int kipp_keep_last_token(int* last_token, long long stride, const int* ids, const int* q_start,
                                    const int* slots, int entries, void* stream) {
    if (entries <= 0) return 0;
    if (last_token == nullptr || stride <= 0) return KIPP_ERR_ARG;
    return kipp_launch(keep_last_token_kernel, dim3((unsigned)((entries + 127) / 128)), dim3(128), 0, (cudaStream_t)stream, 1,
                       last_token, stride, ids, q_start, slots, entries);
}

// ---------------------------------------------------------------------------
// x[r, :] += mult * y[r, :] * rsqrt(mean(y[r, :]^2) + eps) * w: the RMS norm of a sublayer's OUTPUT
// joins the residual stream, all of it float32 (w keeps its storage type).  `copy` (or null) takes
// the new x rounded to bfloat16: the input of the sublayer that reads the stream next.
__global__ void __launch_bounds__(256)
rmsnorm_scaled_add_kernel(float* __restrict__ x, const float* __restrict__ y, const void* __restrict__ w, int w_dtype,
                          int size, float eps, float mult, bf16* __restrict__ copy, int vec) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const float* src = y + (size_t)blockIdx.x * size;
    float* dst = x + (size_t)blockIdx.x * size;
    bf16* cp = copy ? copy + (size_t)blockIdx.x * size : nullptr;
    float ss = 0.f;
    if (vec) {
        // four neighbouring values per thread and step; the order of a row's sum depends on its size only
        for (int i = 4 * threadIdx.x; i < size; i += 4 * blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(src + i);
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (int i = threadIdx.x; i < size; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)size + eps);
    auto weight = [&](int i) {
        return w_dtype == KIPP_DT_F32 ? static_cast<const float*>(w)[i] : to_f32(static_cast<const bf16*>(w)[i]);
    };
    if (vec) {
        for (int i = 4 * threadIdx.x; i < size; i += 4 * blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(src + i);
            float4 o = *reinterpret_cast<const float4*>(dst + i);
            o.x += mult * (v.x * inv * weight(i));
            o.y += mult * (v.y * inv * weight(i + 1));
            o.z += mult * (v.z * inv * weight(i + 2));
            o.w += mult * (v.w * inv * weight(i + 3));
            *reinterpret_cast<float4*>(dst + i) = o;
            if (cp) {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
                uint2 pk;
                pk.x = *reinterpret_cast<const uint32_t*>(&lo);
                pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(cp + i) = pk;
            }
        }
    } else {
        for (int i = threadIdx.x; i < size; i += blockDim.x) {
            const float o = dst[i] + mult * (src[i] * inv * weight(i));
            dst[i] = o;
            if (cp) cp[i] = __float2bfloat16_rn(o);
        }
    }
}

extern "C" int kipp_rmsnorm_scaled_add(float* x, const float* y, const void* w, int w_dtype, int rows, int size, float eps,
                                       float mult, void* copy_bf16, void* stream) {
    if (rows <= 0) return 0;
    if (size <= 0 || !(eps > 0.f) || (w_dtype != KIPP_DT_F32 && w_dtype != KIPP_DT_BF16)) return KIPP_ERR_ARG;
    const int vec = size % 4 == 0 && (((uintptr_t)x | (uintptr_t)y) & 15) == 0 && ((uintptr_t)copy_bf16 & 7) == 0;
    return kipp_launch(rmsnorm_scaled_add_kernel, dim3((unsigned)rows), dim3(size >= 1024 ? 256 : 128), 0, (cudaStream_t)stream,
                       1, x, y, w, w_dtype, size, eps, mult, (bf16*)copy_bf16, vec);
}

// x *= scale over n float32 values (logits of a head with a scale).
__global__ void scale_f32_kernel(float* __restrict__ x, long long n, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] *= scale;
}

extern "C" int kipp_scale_f32(float* x, long long n, float scale, void* stream) {
    if (n <= 0) return 0;
    const long long blocks = (n + 255) / 256;
    if (blocks > 0x7fffffffLL) return KIPP_ERR_ARG;
    return kipp_launch(scale_f32_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, 1, x, n, scale);
}

// ---------------------------------------------------------------------------------------------
// Hyper-connections: the residual stream as S copies x_1 .. x_S, each [tokens, size] float32, `stride`
// floats apart.  One launch does, per token row, up to two things in float32:
//   update (y given)    x_t <- sum_s mix[s * S + t] x_s + mult * out[t] * y      for every t, from the old x_s
//   read (in_w given)   u = sum_s in_w[s] x_s;  h = u * rsqrt(mean(u^2) + eps) * norm_w, in the compute type
// so that the kernel between two sublayers writes the streams once and hands the next sublayer its
// input.  With S = 1 and mix = in = out = 1 this is the plain residual add and pre-norm.
namespace {
constexpr int MAX_STREAMS = 8;
struct HyperArgs {
    float* x; long long stride; int S;
    float* y; int clear_y;
    const float* mix; const float* out_w; float mult;
    const float* in_w; const void* norm_w; int norm_w_dtype; float eps;
    void* h;
    int size;
};

// VEC: values per thread and step (4 where the row's size and the pointers allow 16-byte accesses); MS: the
// most copies this instance holds (4 keeps a thread's values in few enough registers for blocks of 512)
template <typename T, int VEC, int MS>
__global__ void __launch_bounds__(MS <= 4 ? 512 : 256)
hyper_connection_kernel(const HyperArgs a) {
    extern __shared__ __align__(16) float u_row[];        // [size] when the read phase runs
    __shared__ float scratch[32];
    __shared__ float c_mix[MAX_STREAMS * MAX_STREAMS], c_out[MAX_STREAMS], c_in[MAX_STREAMS];
    pdl_launch_dependents();
    pdl_wait();
    const int S = a.S, size = a.size;
    if (threadIdx.x < S * S && a.y != nullptr) c_mix[threadIdx.x] = a.mix ? a.mix[threadIdx.x] : (threadIdx.x % (S + 1) == 0 ? 1.f : 0.f);
    if (threadIdx.x < S) {
        c_out[threadIdx.x] = a.y != nullptr ? a.mult * (a.out_w ? a.out_w[threadIdx.x] : 1.f) : 0.f;
        c_in[threadIdx.x] = a.in_w ? a.in_w[threadIdx.x] : 1.f;
    }
    __syncthreads();
    const bool read = a.h != nullptr;
    float* row = a.x + (size_t)blockIdx.x * size;
    float* yr = a.y ? a.y + (size_t)blockIdx.x * size : nullptr;
    float ss = 0.f;
    for (int i = VEC * threadIdx.x; i < size; i += VEC * blockDim.x) {
        float xs[MS][VEC];
#pragma unroll
        for (int s = 0; s < MS; ++s) {
            if (s >= S) continue;
            if (VEC == 4) *reinterpret_cast<float4*>(xs[s]) = *reinterpret_cast<const float4*>(row + (size_t)s * a.stride + i);
            else xs[s][0] = row[(size_t)s * a.stride + i];
        }
        if (yr != nullptr) {
            float y[VEC], nx[MS][VEC];
            if (VEC == 4) *reinterpret_cast<float4*>(y) = *reinterpret_cast<const float4*>(yr + i);
            else y[0] = yr[i];
            if (a.clear_y) {                            // the next sublayer adds its output into zeros
                if (VEC == 4) *reinterpret_cast<float4*>(yr + i) = make_float4(0.f, 0.f, 0.f, 0.f);
                else yr[i] = 0.f;
            }
#pragma unroll
            for (int t = 0; t < MS; ++t) {
                if (t >= S) continue;
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    float acc = 0.f;
#pragma unroll
                    for (int s = 0; s < MS; ++s)
                        if (s < S) acc = fmaf(c_mix[s * S + t], xs[s][v], acc);
                    nx[t][v] = fmaf(c_out[t], y[v], acc);
                }
            }
#pragma unroll
            for (int t = 0; t < MS; ++t) {
                if (t >= S) continue;
#pragma unroll
                for (int v = 0; v < VEC; ++v) xs[t][v] = nx[t][v];
                if (VEC == 4) *reinterpret_cast<float4*>(row + (size_t)t * a.stride + i) = *reinterpret_cast<const float4*>(nx[t]);
                else row[(size_t)t * a.stride + i] = nx[t][0];
            }
        }
        if (read) {
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                float u = 0.f;
#pragma unroll
                for (int s = 0; s < MS; ++s)
                    if (s < S) u = fmaf(c_in[s], xs[s][v], u);
                u_row[i + v] = u;
                ss = fmaf(u, u, ss);
            }
        }
    }
    if (!read) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)size + a.eps);
    T* h = static_cast<T*>(a.h) + (size_t)blockIdx.x * size;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float w = a.norm_w_dtype == KIPP_DT_F32 ? static_cast<const float*>(a.norm_w)[i]
                                                      : to_f32(static_cast<const bf16*>(a.norm_w)[i]);
        h[i] = from_f32<T>(u_row[i] * inv * w);
    }
}

__global__ void sum_streams_kernel(float* __restrict__ out, const float* __restrict__ x, long long stride, int S,
                                   long long n) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float acc = 0.f;
    for (int s = 0; s < S; ++s) acc += x[(size_t)s * stride + i];
    out[i] = acc;
}
}  // namespace

extern "C" int kipp_hyper_connection_max_streams() { return MAX_STREAMS; }

// y null: no update; h null: no read.  mix [S, S] indexed [from, to], out_w [S], in_w [S] float32 (null: identity / ones).
// clear_y: y is set to zero once it is read (the buffer the next sublayer adds its output into).
extern "C" int kipp_hyper_connection(float* x, long long stride, int streams, float* y, int clear_y, const float* mix,
                                     const float* out_w, float mult, const float* in_w, const void* norm_w,
                                     int norm_w_dtype, float eps, void* h, int h_dtype, int rows, int size, void* stream) {
    if (rows <= 0) return 0;
    if (size <= 0 || streams <= 0 || streams > MAX_STREAMS || x == nullptr) return KIPP_ERR_ARG;
    if (h != nullptr && (norm_w == nullptr || !(eps > 0.f) || (norm_w_dtype != KIPP_DT_F32 && norm_w_dtype != KIPP_DT_BF16)))
        return KIPP_ERR_ARG;
    if ((size_t)size * sizeof(float) > 160 * 1024) return KIPP_ERR_ARG;
    HyperArgs a;
    a.x = x; a.stride = stride; a.S = streams; a.y = y; a.clear_y = clear_y; a.mix = mix; a.out_w = out_w; a.mult = mult;
    a.in_w = in_w; a.norm_w = norm_w; a.norm_w_dtype = norm_w_dtype; a.eps = eps; a.h = h; a.size = size;
    const size_t smem = h != nullptr ? (size_t)size * sizeof(float) : 0;
    const bool vec = size % 4 == 0 && stride % 4 == 0 && (((uintptr_t)x | (uintptr_t)y) & 15) == 0;
    // a thread's steps wait for one another (loads behind stores to the same row): with few rows as few steps
    // as the block allows; with rows enough to fill the GPU several times over, small blocks (measured at
    // 2,048 rows of 4 x 2,048: 36 us with 128 threads, 55 us with 512)
    const int per = vec ? 4 : 1;
    const int wide = std::min(streams <= 4 ? 512 : 256, std::max(64, (size / per + 31) / 32 * 32));
    const dim3 grid((unsigned)rows), block((unsigned)(rows >= 1024 ? std::min(128, wide) : wide));
    auto go = [&](auto kernel) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return kipp_launch(kernel, grid, block, smem, (cudaStream_t)stream, 1, a);
    };
    const bool f32 = h == nullptr || h_dtype == KIPP_DT_F32;
    if (!f32 && h_dtype != KIPP_DT_BF16) return KIPP_ERR_DTYPE;
    if (streams <= 4) {
        if (f32) return vec ? go(hyper_connection_kernel<float, 4, 4>) : go(hyper_connection_kernel<float, 1, 4>);
        return vec ? go(hyper_connection_kernel<bf16, 4, 4>) : go(hyper_connection_kernel<bf16, 1, 4>);
    }
    if (f32) return vec ? go(hyper_connection_kernel<float, 4, MAX_STREAMS>) : go(hyper_connection_kernel<float, 1, MAX_STREAMS>);
    if (h_dtype == KIPP_DT_BF16)
        return vec ? go(hyper_connection_kernel<bf16, 4, MAX_STREAMS>) : go(hyper_connection_kernel<bf16, 1, MAX_STREAMS>);
    return KIPP_ERR_DTYPE;
}

// out[i] = sum_s x[s * stride + i] over n float32 values.
extern "C" int kipp_sum_streams(float* out, const float* x, long long stride, int streams, long long n, void* stream) {
    if (n <= 0) return 0;
    if (streams <= 0) return KIPP_ERR_ARG;
    const long long blocks = (n + 255) / 256;
    if (blocks > 0x7fffffffLL) return KIPP_ERR_ARG;
    return kipp_launch(sum_streams_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, 1, out, x, stride,
                       streams, n);
}

// ---------------------------------------------------------------------------------------------
// A gated feed-forward's activation with limits: g = min(gate + bg, limit), u = clamp(up + bu, -limit, limit),
// out = g * sigmoid(alpha * g) * (u + 1), in float32 from the projection's stored values.  gate of element i
// is proj[r, gate_off + i * step], up proj[r, up_off + i * step].  limit <= 0: no limits.  row_gate given:
// the whole row is also multiplied by sigmoid(row_gate[r]) (a gate per token on the part's output:
// applied here, before the linear down projection).
namespace {
template <typename T>
__global__ void glu_limited_kernel(T* __restrict__ out, long long ld_out, const T* __restrict__ proj, long long ld_proj,
                                   int rows, int n, int gate_off, int up_off, int step, const float* __restrict__ bias_gate,
                                   const float* __restrict__ bias_up, int bias_step, float limit, float alpha,
                                   const float* __restrict__ row_gate) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)rows * n) return;
    const long long r = idx / n;
    const int i = (int)(idx % n);
    const T* pr = proj + r * ld_proj;
    float g = to_f32(pr[gate_off + (long long)i * step]), u = to_f32(pr[up_off + (long long)i * step]);
    if (bias_gate != nullptr) g += bias_gate[(long long)i * bias_step];
    if (bias_up != nullptr) u += bias_up[(long long)i * bias_step];
    if (limit > 0.f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
    }
    float v = g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
    if (row_gate != nullptr) v *= 1.0f / (1.0f + expf(-row_gate[r]));
    out[r * ld_out + i] = from_f32<T>(v);
}

__global__ void add_row_bias_kernel(float* __restrict__ x, const float* __restrict__ bias, long long n, int size) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += bias[i % size];
}

__global__ void softcap_f32_kernel(float* __restrict__ x, long long n, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}
}  // namespace

extern "C" int kipp_glu_limited(void* out, long long ld_out, const void* proj, long long ld_proj, int dtype, int rows, int n,
                                int gate_off, int up_off, int step, const float* bias_gate, const float* bias_up,
                                int bias_step, float limit, float alpha, const float* row_gate, void* stream) {
    if (rows <= 0 || n <= 0) return 0;
    if (step <= 0 || gate_off < 0 || up_off < 0) return KIPP_ERR_ARG;
    const long long total = (long long)rows * n, blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) return KIPP_ERR_ARG;
    if (dtype == KIPP_DT_F32)
        return kipp_launch(glu_limited_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, 1, (float*)out,
                           ld_out, (const float*)proj, ld_proj, rows, n, gate_off, up_off, step, bias_gate, bias_up, bias_step,
                           limit, alpha, row_gate);
    if (dtype == KIPP_DT_BF16)
        return kipp_launch(glu_limited_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, 1, (bf16*)out,
                           ld_out, (const bf16*)proj, ld_proj, rows, n, gate_off, up_off, step, bias_gate, bias_up, bias_step,
                           limit, alpha, row_gate);
    return KIPP_ERR_DTYPE;
}

// out[r] = w . h[r, :] in float32 (w float32 [size]; h in `dtype`): a block per row, the order of the sum
// fixed by the size.
namespace {
template <typename T>
__global__ void __launch_bounds__(128)
row_dot_kernel(float* __restrict__ out, const T* __restrict__ h, long long ldh, const float* __restrict__ w, int rows, int size) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const T* row = h + (size_t)blockIdx.x * ldh;
    float acc = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) acc = fmaf(w[i], to_f32(row[i]), acc);
    acc = block_sum(acc, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = acc;
}
}  // namespace
extern "C" int kipp_row_dot(float* out, const void* h, long long ldh, int dtype, const float* w, int rows, int size, void* stream) {
    if (rows <= 0) return 0;
    if (size <= 0 || w == nullptr) return KIPP_ERR_ARG;
    const dim3 grid((unsigned)rows);
    if (dtype == KIPP_DT_F32)
        return kipp_launch(row_dot_kernel<float>, grid, dim3(128), 0, (cudaStream_t)stream, 1, out, (const float*)h, ldh, w, rows, size);
    if (dtype == KIPP_DT_BF16)
        return kipp_launch(row_dot_kernel<bf16>, grid, dim3(128), 0, (cudaStream_t)stream, 1, out, (const bf16*)h, ldh, w, rows, size);
    return KIPP_ERR_DTYPE;
}

// x[r, :] += bias over rows of `size` float32 values.
extern "C" int kipp_add_row_bias(float* x, const float* bias, int rows, int size, void* stream) {
    if (rows <= 0 || size <= 0) return 0;
    const long long n = (long long)rows * size, blocks = (n + 255) / 256;
    if (blocks > 0x7fffffffLL || bias == nullptr) return KIPP_ERR_ARG;
    return kipp_launch(add_row_bias_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, 1, x, bias, n, size);
}

// x <- cap * tanh(x / cap) over n float32 values (logits with a soft cap).
extern "C" int kipp_softcap_f32(float* x, long long n, float cap, void* stream) {
    if (n <= 0) return 0;
    const long long blocks = (n + 255) / 256;
    if (blocks > 0x7fffffffLL || !(cap > 0.f)) return KIPP_ERR_ARG;
    return kipp_launch(softcap_f32_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, 1, x, n, cap);
}
